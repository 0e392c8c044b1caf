"""Tensor caches: latents and text embeddings keyed by content.

Values use the reference's headered tensor format `KMT1`
(`src/kohakumoss_data/cache/store.py:19-112`): `<4sBBHf` = magic, dtype code (1 bf16, 2 fp16,
3 fp32, 4 fp8 e4m3 with one fp32 scale), ndim, 0, scale; then ndim u32 dims; then raw bytes.
Keys are the blake2b-128 hashes of `src/kohakumoss_data/cache/keys.py:7-35` (every input that
changes the tensor takes part).

The container is not a database: a store is an append-only data file `<stem>.kmts` plus an
index `<stem>.kmti` of 32-byte records (16-byte key, u64 offset, u32 bytes, u32 first dim).
Readers map the data file and slice values out of the page cache without a copy until the
dtype conversion; the index is one `np.fromfile`. One writer per file: the offline build
writes the main file; each online writer (rank r) appends to its own `<stem>.r<r>.kmts`
shard and readers see every shard; `merge_shards` folds them into the main file.
"""

from __future__ import annotations

import glob
import hashlib
import os
import struct
import threading

import numpy as np
import torch
from torch import Tensor

MAGIC = b"KMT1"
HEAD = struct.Struct("<4sBBHf")
STORAGE = {"bf16": (1, torch.bfloat16), "fp16": (2, torch.float16), "fp32": (3, torch.float32), "fp8": (4, torch.float8_e4m3fn)}
CODES = {code: (name, dt) for name, (code, dt) in STORAGE.items()}
FP8_MAX = 448.0
MODES = ("off", "offline", "online")
INDEX = np.dtype([("key", "S16"), ("offset", "<u8"), ("size", "<u4"), ("first", "<u4")])


def text_hash(*parts) -> str:
    return hashlib.blake2b("\x1f".join(str(p) for p in parts).encode("utf-8"), digest_size=16).hexdigest()


def content_hash(data: bytes) -> str:
    return hashlib.blake2b(data, digest_size=16).hexdigest()


def latent_key(row, item, encoder_id: str, dtype: str, background: str, resample: str = "lanczos", draw: str = "mode") -> str:
    content = row.extra.get("hash") or f"{row.locator}:{row.w}x{row.h}"
    return text_hash("latent", content, encoder_id, dtype, tuple(item.target_hw), tuple(item.crop_ltrb), int(item.flip),
                     background if row.has_alpha else "", resample, draw)


def text_key(caption: str, encoder_id: str, dtype: str) -> str:
    return text_hash("text", encoder_id, dtype, caption)


# ---- value format ------------------------------------------------------------------------------
def fp8_scale(t: Tensor) -> Tensor:
    amax = t.detach().float().abs().amax() if t.numel() else t.new_zeros(())
    return torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax)).float()


def encode_tensor(t: Tensor, storage: str) -> bytes:
    code, dtype = STORAGE[storage]
    t = t.detach().to("cpu").contiguous()
    scale = 1.0
    if storage == "fp8":
        t = t.float()
        s = fp8_scale(t)
        scale, payload = float(s), (t / s).to(dtype)
    else:
        payload = t.to(dtype)
    raw = payload.view(torch.uint8).numpy().tobytes()
    return HEAD.pack(MAGIC, code, t.ndim, 0, scale) + struct.pack(f"<{t.ndim}I", *t.shape) + raw


def _header(data) -> tuple[int, float, tuple[int, ...], int]:
    magic, code, ndim, _, scale = HEAD.unpack_from(data, 0)
    if magic != MAGIC:
        raise ValueError("not a tensor-store value")
    shape = struct.unpack_from(f"<{ndim}I", data, HEAD.size)
    return code, scale, shape, HEAD.size + 4 * ndim


def decode_tensor(data, out_dtype: torch.dtype = torch.bfloat16) -> Tensor:
    code, scale, shape, off = _header(data)
    _, dtype = CODES[code]
    buf = np.frombuffer(data, dtype=np.uint8, offset=off).copy()
    t = torch.from_numpy(buf).view(dtype).reshape(shape)
    return (t.float() * scale).to(out_dtype) if code == 4 else t.to(out_dtype)


def stored_value(t: Tensor, storage: str, out_dtype: torch.dtype = torch.bfloat16) -> Tensor:
    """What a store round trip returns, computed on `t`'s device (bit-identical)."""
    _, dtype = STORAGE[storage]
    if storage == "fp8":
        s = fp8_scale(t)
        return ((t.detach().float() / s).to(dtype).float() * s).to(out_dtype)
    return t.detach().to(dtype).to(out_dtype)


class LengthTable:
    """Sorted 16-byte keys -> first-dim lengths (compact, cheap to pickle)."""

    def __init__(self, keys: np.ndarray | None = None, lens: np.ndarray | None = None):
        self.keys = np.empty(0, dtype="S16") if keys is None else keys
        self.lens = np.empty(0, dtype=np.int32) if lens is None else lens

    def get(self, key: str) -> int | None:
        k = np.array(bytes.fromhex(key), dtype="S16")
        i = int(np.searchsorted(self.keys, k))
        # numpy strips trailing NULs of S16 values on both sides, so equal keys compare equal
        return int(self.lens[i]) if i < len(self.keys) and self.keys[i] == k else None

    def __len__(self) -> int:
        return len(self.keys)


class _File:
    """One (data, index) pair opened for reading; reloads when the index grew."""

    def __init__(self, stem: str):
        self.stem = stem
        self.size = -1
        self.index: dict[bytes, tuple[int, int, int]] = {}
        self.map = None
        self.refresh()

    def refresh(self) -> None:
        ipath = self.stem + ".kmti"
        size = os.path.getsize(ipath) if os.path.exists(ipath) else 0
        if size == self.size:
            return
        usable = size // INDEX.itemsize
        rec = np.fromfile(ipath, dtype=INDEX, count=usable) if usable else np.empty(0, dtype=INDEX)
        self.records = rec
        self.index = {bytes(r["key"]).ljust(16, b"\0"): (int(r["offset"]), int(r["size"]), int(r["first"])) for r in rec}
        self.map = np.memmap(self.stem + ".kmts", dtype=np.uint8, mode="r") if usable else None
        self.size = size

    def get(self, key: bytes):
        hit = self.index.get(key)
        if hit is None or self.map is None:
            return None
        off, size, _ = hit
        if off + size > self.map.shape[0]:
            self.map = np.memmap(self.stem + ".kmts", dtype=np.uint8, mode="r")
        return self.map[off : off + size]


class TensorStore:
    def __init__(self, path: str, storage: str = "bf16", writer_rank: int | None = None):
        """`path` names the main file stem (any extension is dropped). `writer_rank=None` writes
        the main file (offline build); an int writes that rank's shard."""
        self.stem = os.path.splitext(path)[0]
        self.storage = storage
        self.writer_rank = writer_rank
        self._files: dict[str, _File] = {}
        self._out = None
        self._lock = threading.Lock()
        self._scan()

    def __getstate__(self):
        return {"stem": self.stem, "storage": self.storage, "writer_rank": self.writer_rank}

    def __setstate__(self, s):
        self.__dict__.update(s)
        self._files, self._out, self._lock = {}, None, threading.Lock()
        self._scan()

    def _scan(self) -> None:
        stems = [self.stem] + sorted(os.path.splitext(p)[0] for p in glob.glob(glob.escape(self.stem) + ".r*.kmti"))
        for s in stems:
            if s in self._files:
                self._files[s].refresh()
            elif os.path.exists(s + ".kmti"):
                self._files[s] = _File(s)

    def refresh(self) -> None:
        self._scan()

    def _raw(self, key: str):
        k = bytes.fromhex(key)
        for f in self._files.values():
            hit = f.get(k)
            if hit is not None:
                return hit
        return None

    def get(self, key: str, out_dtype: torch.dtype = torch.bfloat16) -> Tensor | None:
        raw = self._raw(key)
        return None if raw is None else decode_tensor(raw, out_dtype)

    def __contains__(self, key: str) -> bool:
        k = bytes.fromhex(key)
        return any(k in f.index for f in self._files.values())

    def __len__(self) -> int:
        return len({k for f in self._files.values() for k in f.index})

    def lengths(self) -> LengthTable:
        merged: dict[bytes, int] = {}
        for f in self._files.values():
            for k, (_, _, first) in f.index.items():
                merged[k] = first
        keys = np.array(sorted(merged), dtype="S16")
        lens = np.array([merged[k] for k in sorted(merged)], dtype=np.int32)
        return LengthTable(keys, lens)

    # -- writing --------------------------------------------------------------------------------
    def _writer_stem(self) -> str:
        return self.stem if self.writer_rank is None else f"{self.stem}.r{self.writer_rank}"

    def put(self, key: str, t: Tensor) -> None:
        """Append one value (data first, then its index record, so a reader never sees an index
        record without data). A key that is already present is skipped."""
        if key in self:
            return
        data = encode_tensor(t, self.storage)
        with self._lock:
            stem = self._writer_stem()
            if self._out is None:
                os.makedirs(os.path.dirname(os.path.abspath(stem)), exist_ok=True)
                self._out = (open(stem + ".kmts", "ab"), open(stem + ".kmti", "ab"))
            d, i = self._out
            off = d.seek(0, os.SEEK_END)
            pad = (-off) % 64
            if pad:
                d.write(b"\0" * pad)
                off += pad
            d.write(data)
            d.flush()
            rec = np.zeros(1, dtype=INDEX)
            rec["key"], rec["offset"], rec["size"], rec["first"] = bytes.fromhex(key), off, len(data), int(t.shape[0]) if t.ndim else 1
            i.write(rec.tobytes())
            i.flush()
        self._scan()

    def close(self) -> None:
        with self._lock:
            if self._out is not None:
                for f in self._out:
                    f.close()
                self._out = None


def merge_shards(path: str, storage: str = "bf16", remove: bool = True) -> int:
    """Fold every `<stem>.r<rank>` shard into the main file; returns the values moved."""
    stem = os.path.splitext(path)[0]
    main = TensorStore(stem, storage)
    moved = 0
    for ipath in sorted(glob.glob(glob.escape(stem) + ".r*.kmti")):
        shard = _File(os.path.splitext(ipath)[0])
        for key in list(shard.index):
            hexkey = key.hex()
            if hexkey in _MainOnly(main):
                continue
            raw = shard.get(key)
            _append_raw(main, hexkey, bytes(raw), shard.index[key][2])
            moved += 1
        if remove:
            shard.map = None
            os.remove(shard.stem + ".kmti")
            os.remove(shard.stem + ".kmts")
    main.close()
    return moved


class _MainOnly:
    def __init__(self, store: TensorStore):
        self.file = store._files.get(store.stem)

    def __contains__(self, key: str) -> bool:
        return self.file is not None and bytes.fromhex(key) in self.file.index


def _append_raw(store: TensorStore, key: str, data: bytes, first: int) -> None:
    stem = store.stem
    if store._out is None:
        store._out = (open(stem + ".kmts", "ab"), open(stem + ".kmti", "ab"))
    d, i = store._out
    off = d.seek(0, os.SEEK_END)
    pad = (-off) % 64
    d.write(b"\0" * pad + data)
    d.flush()
    rec = np.zeros(1, dtype=INDEX)
    rec["key"], rec["offset"], rec["size"], rec["first"] = bytes.fromhex(key), off + pad, len(data), first
    i.write(rec.tobytes())
    i.flush()
    if store._files.get(stem) is None:
        store._files[stem] = _File(stem)
    else:
        store._files[stem].refresh()


class _Cache:
    def __init__(self, path: str | None, mode: str, encoder_id: str, storage: str, writer_rank: int | None = None):
        if mode not in MODES:
            raise ValueError(f"cache mode must be one of {MODES}, got {mode}")
        if mode != "off" and not path:
            raise ValueError(f"cache mode {mode} needs a path")
        self.mode, self.encoder_id, self.storage = mode, encoder_id, storage
        self.store = TensorStore(path, storage, writer_rank if mode == "online" else None) if mode != "off" else None

    @property
    def enabled(self) -> bool:
        return self.store is not None

    def get(self, key: str, out_dtype=torch.bfloat16):
        return None if self.store is None else self.store.get(key, out_dtype)

    def put(self, key: str, t: Tensor) -> None:
        if self.store is not None:
            self.store.put(key, t)

    def lengths(self) -> LengthTable:
        return LengthTable() if self.store is None else self.store.lengths()


class LatentCache(_Cache):
    """Packed latent tokens `[h * w, C]` per (image, geometry, flip, decode options)."""

    def __init__(self, path, mode="off", encoder_id="", storage="bf16", background="white", resample="lanczos", draw="mode", writer_rank=None):
        super().__init__(path, mode, encoder_id, storage, writer_rank)
        self.background, self.resample, self.draw = background, resample, draw

    def key(self, row, item) -> str:
        return latent_key(row, item, self.encoder_id, self.storage, self.background, self.resample, self.draw)

    def as_cached(self, full: Tensor, hw: Tensor, out_dtype=torch.bfloat16) -> Tensor:
        sizes = (hw[:, 0].long() * hw[:, 1].long()).tolist()
        return torch.cat([stored_value(p, self.storage, out_dtype) for p in full.split(sizes, 0)], 0)


class TextCache(_Cache):
    """Unpadded text embeddings `[L, D]` per rendered caption."""

    def key(self, caption: str) -> str:
        return text_key(caption, self.encoder_id, self.storage)

    def as_cached(self, parts: list[Tensor], out_dtype=torch.bfloat16) -> list[Tensor]:
        return [stored_value(p, self.storage, out_dtype) for p in parts]
