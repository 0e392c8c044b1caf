"""MossDataset: sources + catalog + captions + planner + caches -> `HostBatch` per index.

`materialize(index, rank, world)` is a pure function (picklable object, no iteration state), so
the loader is stateless and a resumed run replays the same batches. Roles and knob semantics
follow the reference dataset and data config (`src/kohakumoss_data/dataset.py:142-456`,
`config.py:20-209`): cache modes `off | offline | online` for latents and text, token budgets
`estimate | render | exact`, seeded caption dropout, per-dataset loss weights, over-long fits.
"""

from __future__ import annotations

import fcntl
import io
import math
import os
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from ..utils.log import get_logger
from .captions import CAPTIONS, bind_template, build_template
from .catalog import Catalog, is_catalog, merge_scan
from .geometry import LATENT_FACTOR, Geometry
from .planner import BATCHINGS, OVERLONG, PLANNERS, keep_indices, rng_of
from .sources import SOURCES, build_source
from .store import MODES, STORAGE, LatentCache, LengthTable, TextCache, text_hash
from .types import HostBatch

log = get_logger("data")
TOKEN_BUDGETS = ("estimate", "render", "exact")
BACKGROUNDS = {"white": (255, 255, 255), "black": (0, 0, 0), "gray": (127, 127, 127)}
RESAMPLE = ("lanczos", "bicubic", "bilinear", "box")
RESCAN = (False, True, "full")


@dataclass
class DataConfig:
    """Every data knob (lower-case names of the train-script globals)."""

    datasets: list = field(default_factory=list)
    resolution_mode: str = "resize"
    target_area: int = 1024 * 1024
    size_step: int = 16
    aspect_range: tuple = (0.25, 4.0)
    upscale: str = "never"
    crop: str = "center"
    batching: str = "tokens"
    max_tokens: int = 16384
    max_samples: int = 0
    token_budget: str = "estimate"
    overlong: str = "drop"
    batch_size: int = 4
    planner_kwargs: dict = field(default_factory=dict)
    caption: dict = field(default_factory=lambda: {"template": "tags"})
    caption_variants: int = 4
    text_drop: float = 0.1
    latent_cache: str = "offline"
    text_cache: str = "offline"
    cache_dtype: str = "bf16"
    cache_dir: str = ""
    latent_encoder_id: str = "flux2-vae"
    latent_encoder_spec: str = ""
    latent_draw: str = "mode"
    text_encoder_id: str = "qwen3.5-9b"
    text_encoder_spec: str = ""
    latent_factor: int = LATENT_FACTOR
    flip: bool = False
    background: object = "white"
    resample: str = "lanczos"
    text_chars_per_token: float = 3.5
    text_overhead_tokens: int = 12
    max_text_tokens: int = 4096
    num_workers: int = 4
    prefetch: int = 2
    pin_memory: bool = True
    seed: int = 0
    data_rescan: object = False
    data_scan_workers: int = 8
    data_wait: float = 3600.0
    data_balance: bool = False
    grad_acc: int = 1

    @classmethod
    def from_knobs(cls, knobs: dict) -> "DataConfig":
        names = cls.__dataclass_fields__
        picked = {k.lower(): v for k, v in knobs.items() if k.lower() in names}
        for k in ("latent_encoder_id", "text_encoder_id"):
            if picked.get(k) == "":
                picked.pop(k)
        if not picked.get("caption"):
            picked.pop("caption", None)
        cfg = cls(**picked)
        cfg.cache_dir = resolved_cache_dir(cfg)
        return cfg


def _default_cache_dir(cfg: DataConfig) -> str:
    paths = [str(e["path"]) for e in cfg.datasets if e.get("path")]
    if not paths:
        return ""
    p = paths[0]
    is_file = "*" in p or os.path.isfile(p) or bool(os.path.splitext(p)[1])
    return os.path.join(os.path.dirname(os.path.abspath(p)) if is_file else p, "cache")


def resolved_cache_dir(cfg: DataConfig) -> str:
    if cfg.cache_dir:
        return cfg.cache_dir
    if cfg.latent_cache == "off" and cfg.text_cache == "off":
        return ""
    return _default_cache_dir(cfg)


def catalog_cache_dir(cfg: DataConfig) -> str:
    return cfg.cache_dir or _default_cache_dir(cfg)


def encoder_key_id(encoder_id: str, spec: str) -> str:
    return f"{encoder_id}/{spec}" if spec else encoder_id


def data_problems(cfg: DataConfig) -> list[str]:
    """Every knob combination that would make the dataset (or its first batch) fail."""
    out = []
    for name, value, allowed in (
        ("RESOLUTION_MODE", cfg.resolution_mode, PLANNERS.names()), ("BATCHING", cfg.batching, sorted(BATCHINGS)),
        ("OVERLONG", cfg.overlong, sorted(OVERLONG)), ("LATENT_CACHE", cfg.latent_cache, list(MODES)),
        ("TEXT_CACHE", cfg.text_cache, list(MODES)), ("CACHE_DTYPE", cfg.cache_dtype, sorted(STORAGE)),
        ("TOKEN_BUDGET", cfg.token_budget, list(TOKEN_BUDGETS)), ("DATA_RESCAN", cfg.data_rescan, list(RESCAN)),
        ("UPSCALE", cfg.upscale, ["never", "to_area"]), ("CROP", cfg.crop, ["center", "random"]),
        ("LATENT_DRAW", cfg.latent_draw, ["mode", "sample"]), ("RESAMPLE", cfg.resample, sorted(RESAMPLE)),
    ):
        if value not in allowed:
            out.append(f"{name}={value!r} is not one of {list(allowed)}")
    if isinstance(cfg.background, str) and cfg.background not in BACKGROUNDS:
        out.append(f"BACKGROUND={cfg.background!r} is not one of {sorted(BACKGROUNDS)}")
    if not cfg.datasets:
        out.append("DATASETS is empty")
    if (cfg.latent_cache != "off" or cfg.text_cache != "off") and not resolved_cache_dir(cfg):
        out.append("a cache is not 'off' but CACHE_DIR is empty and no dataset has a path: set CACHE_DIR")
    if cfg.token_budget == "exact" and cfg.text_cache != "offline":
        out.append("TOKEN_BUDGET='exact' needs TEXT_CACHE='offline'")
    random_crop = cfg.crop == "random" or cfg.resolution_mode == "shifted_square"
    if cfg.latent_cache == "offline" and random_crop:
        out.append("LATENT_CACHE='offline' needs a centre crop (CROP='center', not RESOLUTION_MODE='shifted_square')")
    if cfg.size_step % cfg.latent_factor:
        out.append(f"SIZE_STEP must be a multiple of the latent factor ({cfg.latent_factor})")
    if cfg.max_tokens < 2:
        out.append("MAX_TOKENS must be >= 2")
    for entry in cfg.datasets:
        name = entry.get("source") or entry.get("type")
        if name not in SOURCES:
            out.append(f"dataset source {name!r} is not one of {list(SOURCES.names())}")
            continue
        src = SOURCES.get(name)
        if hasattr(src, "problems"):
            out += src.problems(entry)
        cap = entry.get("caption", cfg.caption) or {}
        kind = cap.get("template", "tags") if isinstance(cap, dict) else cap
        tmpl = CAPTIONS.get(kind) if kind in CAPTIONS else None
        if getattr(tmpl, "geometric", False) and (random_crop or cfg.flip):
            out.append(f"caption template {kind!r} follows the row's centre crop: needs CROP='center', FLIP=False "
                       "and not RESOLUTION_MODE='shifted_square'")
    return out


def pipeline_problems(cfg: DataConfig) -> list[str]:
    """What keeps every planned batch from fitting a static pipeline micro-batch shape."""
    out = []
    if cfg.batching == "count":
        out.append("pipeline needs BATCHING='tokens' or 'tokens_ffd', not 'count'")
    if cfg.max_samples < 1:
        out.append("pipeline needs MAX_SAMPLES >= 1 (the micro-batch sample slots)")
    return out


# ---- decode ------------------------------------------------------------------------------------
class Decoder:
    """bytes -> uint8 [H, W, 3]: EXIF orientation, crop, alpha over background, resize, flip."""

    def __init__(self, background="white", resample: str = "lanczos"):
        self.background = BACKGROUNDS[background] if isinstance(background, str) else tuple(int(c) for c in background)
        self.resample = resample

    def __call__(self, data: bytes, crop_ltrb, target_hw, flip: bool) -> np.ndarray:
        from PIL import Image, ImageOps

        with Image.open(io.BytesIO(data)) as raw:
            ImageOps.exif_transpose(raw, in_place=True)
            img = raw.crop(tuple(crop_ltrb))
            if img.mode in ("RGBA", "LA", "PA", "RGBa", "La") or (img.mode == "P" and "transparency" in img.info):
                rgba = img.convert("RGBA")
                base = Image.new("RGBA", rgba.size, self.background + (255,))
                img = Image.alpha_composite(base, rgba).convert("RGB")
            else:
                img = img.convert("RGB")
        th, tw = target_hw
        if img.size != (tw, th):
            img = img.resize((tw, th), getattr(Image.Resampling, self.resample.upper()), reducing_gap=3.0)
        if flip:
            img = img.transpose(Image.Transpose.FLIP_LEFT_RIGHT)
        return np.array(img, dtype=np.uint8)


# ---- catalog scan with a single writer -----------------------------------------------------------
def scan_path(cache_dir: str, entry_kwargs: dict) -> str:
    return os.path.join(cache_dir, "catalog-" + text_hash(sorted((k, str(v)) for k, v in entry_kwargs.items()))[:16] + ".kmc")


def scan_source(entry: dict, source, cfg: DataConfig, writer: bool = True) -> Catalog:
    """Catalog of one dataset entry: its prebuilt `catalog` file, the source's own catalog, or a
    scan cached in the catalog cache dir. Only the `writer` process scans and writes (under an
    exclusive lock file); the others wait up to `data_wait` seconds for the file to appear."""
    prebuilt = entry.get("catalog")
    if prebuilt and is_catalog(prebuilt):
        return Catalog.load(prebuilt)
    if getattr(source, "catalog", None) is not None:
        return source.catalog()
    cache_dir = catalog_cache_dir(cfg)
    kwargs = {k: v for k, v in entry.items() if k not in ("weight", "caption", "loss_weight", "catalog", "import_to")}
    target = scan_path(cache_dir, kwargs) if cache_dir else None
    if target is None:
        return Catalog(source.scan())
    if not writer:
        deadline = time.time() + cfg.data_wait
        while not is_catalog(target):
            if time.time() > deadline:
                raise TimeoutError(f"waited {cfg.data_wait}s for the catalog writer to produce {target}")
            time.sleep(0.2)
        return Catalog.load(target)
    os.makedirs(cache_dir, exist_ok=True)
    with open(target + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            old = Catalog.load(target) if is_catalog(target) else None
            if old is not None and cfg.data_rescan is False:
                return old
            if hasattr(source, "workers"):
                source.workers = cfg.data_scan_workers
            found = source.scan()
            cat, stats = merge_scan(None if cfg.data_rescan == "full" else old, found)
            cat.save(target)
            log.info(f"catalog {os.path.basename(target)}: {len(cat)} rows ({stats})")
            return Catalog.load(target)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


@dataclass(frozen=True)
class RowGeometry:
    w: int
    h: int
    target_hw: tuple
    crop_ltrb: tuple


class _ColumnLen:
    """Text length from the estimate column (callable per row, vectorised with `many`)."""

    def __init__(self, est: np.ndarray):
        self.est = est

    def __call__(self, row_id: int, variant: int) -> int:
        return int(self.est[row_id])

    def many(self, rows: np.ndarray) -> np.ndarray:
        return self.est[rows]


class MossDataset:
    def __init__(self, cfg: DataConfig, writer: bool = True, rank: int | None = None):
        if not cfg.datasets:
            raise ValueError("DATASETS is empty")
        problems = data_problems(cfg)
        if problems:
            raise ValueError("data config: " + "; ".join(problems))
        self.cfg = cfg
        self.sources = [build_source(e) for e in cfg.datasets]
        parts = [scan_source(e, s, cfg, writer) for e, s in zip(cfg.datasets, self.sources)]
        self.catalog = Catalog.concat(parts, [float(e.get("weight", 1.0)) for e in cfg.datasets])
        self.templates = [build_template(e.get("caption", cfg.caption)) for e in cfg.datasets]
        self.loss_weight = np.array([float(e.get("loss_weight", 1.0)) for e in cfg.datasets], dtype=np.float32)
        self._text_est = self._estimate_columns()
        cache_dir = resolved_cache_dir(cfg)
        self.latents = LatentCache(os.path.join(cache_dir, "latents") if cache_dir else None, cfg.latent_cache,
                                   encoder_key_id(cfg.latent_encoder_id, cfg.latent_encoder_spec), cfg.cache_dtype,
                                   str(cfg.background), cfg.resample, cfg.latent_draw, writer_rank=rank)
        self.texts = TextCache(os.path.join(cache_dir, "text") if cache_dir else None, cfg.text_cache,
                               encoder_key_id(cfg.text_encoder_id, cfg.text_encoder_spec), cfg.cache_dtype, writer_rank=rank)
        self.geometry = Geometry(cfg.target_area, cfg.size_step, tuple(cfg.aspect_range), cfg.upscale, cfg.crop, cfg.latent_factor)
        self.decode = Decoder(cfg.background, cfg.resample)
        self._text_lengths = self.texts.lengths() if cfg.text_cache == "offline" else LengthTable()
        self.planner = self._planner()
        budget = int(max(cfg.max_text_tokens - cfg.text_overhead_tokens, 1) * cfg.text_chars_per_token)
        self.renderers = [bind_template(t, s, self.row_geometry, budget) for t, s in zip(self.templates, self.sources)]

    # -- text lengths ---------------------------------------------------------------------------
    def _estimate_columns(self) -> np.ndarray:
        cfg, cat = self.cfg, self.catalog
        chars = np.zeros(len(cat), dtype=np.int64)
        for k, t in enumerate(self.templates):
            rows = cat.source == k
            est = t.estimate_chars(cat) if hasattr(t, "estimate_chars") else sum(cat.chars.values())
            chars[rows] = est[rows]
        tokens = np.ceil(chars.astype(np.float32) / np.float32(cfg.text_chars_per_token)).astype(np.int64)
        return np.minimum(tokens + cfg.text_overhead_tokens, cfg.max_text_tokens)

    def estimate_text_tokens(self, caption: str) -> int:
        n = math.ceil(len(caption) / self.cfg.text_chars_per_token)
        return min(n + self.cfg.text_overhead_tokens, self.cfg.max_text_tokens)

    def text_len(self, row_id: int, variant: int) -> int:
        mode = self.cfg.token_budget
        if mode == "estimate":
            return int(self._text_est[row_id])
        caption = self.caption(row_id, variant)
        known = self._text_lengths.get(self.texts.key(caption)) if len(self._text_lengths) else None
        if known is not None:
            return known
        if mode == "exact":
            raise KeyError(f"token_budget='exact': caption of row {row_id} variant {variant} is not in the text cache; "
                           "run scripts/data/cache_text.py")
        return self.estimate_text_tokens(caption)

    def _planner(self):
        cfg = self.cfg
        text_len = _ColumnLen(self._text_est) if cfg.token_budget == "estimate" else self.text_len
        kw = dict(catalog=self.catalog, geometry=self.geometry, seed=cfg.seed, flip=cfg.flip, caption_variants=cfg.caption_variants,
                  text_len=text_len, batching=cfg.batching, overlong=cfg.overlong, max_tokens=cfg.max_tokens,
                  max_samples=cfg.max_samples, batch_size=cfg.batch_size, balance=cfg.grad_acc if cfg.data_balance else 0)
        kw.update(cfg.planner_kwargs)
        return PLANNERS.get(cfg.resolution_mode)(**kw)

    # -- rows -----------------------------------------------------------------------------------
    def caption(self, row_id: int, variant: int) -> str:
        row = self.catalog[row_id]
        render = self.renderers[int(self.catalog.source[row_id])]
        return render(row, rng_of("caption", self.cfg.seed, row_id, variant), row_id)

    def row_geometry(self, row_id: int) -> RowGeometry:
        w, h = int(self.catalog.w[row_id]), int(self.catalog.h[row_id])
        target = tuple(int(v) for v in self.planner.targets[row_id])
        return RowGeometry(w, h, target, self.geometry.center_box(w, h, target))

    def open(self, row_id: int) -> bytes:
        return self.sources[int(self.catalog.source[row_id])].open(self.catalog.locator(row_id))

    def pixels(self, item) -> np.ndarray:
        return self.decode(self.open(item.row_id), item.crop_ltrb, item.target_hw, item.flip)

    def __len__(self) -> int:
        return self.planner.epoch_length(0)

    # -- batches --------------------------------------------------------------------------------
    def materialize(self, index: int, rank: int = 0, world: int = 1, pin: bool = False) -> HostBatch:
        cfg = self.cfg
        items = self.planner.plan(index, rank, world).items
        lf = cfg.latent_factor
        drops = [bool(cfg.text_drop) and bool(rng_of("text-drop", cfg.seed, index, rank, slot).random() < cfg.text_drop)
                 for slot in range(len(items))]
        captions = ["" if d else self.caption(it.row_id, it.caption_variant) for it, d in zip(items, drops)]
        ids = [it.row_id for it in items]
        grid = [(it.target_hw[0] // lf, it.target_hw[1] // lf) for it in items]
        keeps = [keep_indices(it, h * w) for it, (h, w) in zip(items, grid)]
        batch = HostBatch(
            latents=None, text=None, hw=torch.tensor(grid, dtype=torch.int32), text_len=torch.zeros(len(items), dtype=torch.int32),
            index=index, ids=torch.tensor(ids, dtype=torch.int64), text_drop=torch.tensor(drops, dtype=torch.bool),
            weight=torch.from_numpy(self.loss_weight[self.catalog.source[ids]].astype(np.float32)),
            img_keep=[None if k is None else torch.from_numpy(k) for k in keeps], rank=rank, text_limit=[it.text_limit for it in items])
        self._fill_latents(batch, items)
        self._fill_text(batch, captions)
        if batch.encoded:
            batch.finalize()
            if pin:
                batch.pin_memory()
        return batch

    def _fill_latents(self, batch: HostBatch, items) -> None:
        mode = self.cfg.latent_cache
        if mode != "off":
            keys = [self.latents.key(self.catalog[it.row_id], it) for it in items]
            batch.latent_keys = keys
            found = [self.latents.get(k) for k in keys]
            missing = [i for i, t in enumerate(found) if t is None]
            if not missing:
                batch.latents = torch.cat([t if k is None else t.index_select(0, k) for t, k in zip(found, batch.img_keep)])
                return
            if mode == "offline":
                it = items[missing[0]]
                raise KeyError(f"latent cache (offline) misses {len(missing)} of {len(items)} samples; first: row {it.row_id} "
                               f"{self.catalog.locator(it.row_id)} -> target {it.target_hw[1]}x{it.target_hw[0]} crop {it.crop_ltrb} "
                               f"flip {it.flip}; run scripts/data/cache_latents.py or set LATENT_CACHE='online'")
        batch.pixels = [torch.from_numpy(self.pixels(it)) for it in items]

    def _fill_text(self, batch: HostBatch, captions: list[str]) -> None:
        mode = self.cfg.text_cache
        if mode != "off":
            keys = [self.texts.key(c) for c in captions]
            batch.text_keys = keys
            found = [self.texts.get(k) for k in keys]
            missing = [i for i, t in enumerate(found) if t is None]
            if not missing:
                set_text(batch, found)
                return
            if mode == "offline":
                raise KeyError(f"text cache (offline) misses {len(missing)} of {len(captions)} captions; first: "
                               f"{captions[missing[0]][:80]!r}; run scripts/data/cache_text.py or set TEXT_CACHE='online'")
        batch.prompts = captions

    def write_back(self, batch: HostBatch, latents=None, text=None) -> None:
        """Online caches: store the trainer's encodings of a batch under its keys (`latents`
        packed full-grid [N_img, C] in batch order; `text` one tensor per sample)."""
        if latents is not None and self.cfg.latent_cache == "online" and batch.latent_keys:
            sizes = (batch.hw[:, 0].long() * batch.hw[:, 1].long()).tolist()
            for key, part in zip(batch.latent_keys, latents.split(sizes)):
                self.latents.put(key, part)
        if text is not None and self.cfg.text_cache == "online" and batch.text_keys:
            for key, emb in zip(batch.text_keys, text):
                self.texts.put(key, emb)


def set_text(batch: HostBatch, found: list) -> None:
    cut = [t[: limit or None] for t, limit in zip(found, batch.text_limit)]
    batch.text = torch.cat(cut)
    batch.text_len = torch.tensor([t.shape[0] for t in cut], dtype=torch.int32)


def encode_missing(batch: HostBatch, dataset: MossDataset | None, encode_images=None, encode_text=None) -> HostBatch:
    """Fill what the caches did not have: `encode_images(pixels, hw) -> [N_img, C]` (full grids)
    and `encode_text(prompts) -> list[[L_i, D]]`, write the results back to online caches, apply
    the over-long fits and build the layout."""
    if batch.latents is None:
        if encode_images is None:
            raise RuntimeError("batch has pixels but no image encoder is bound (set VAE, or build the latent cache)")
        full = encode_images(batch.pixels, batch.hw).detach().to("cpu")
        if dataset is not None:
            dataset.write_back(batch, latents=full)
            full = dataset.latents.as_cached(full, batch.hw, full.dtype) if dataset.latents.enabled else full
        sizes = (batch.hw[:, 0].long() * batch.hw[:, 1].long()).tolist()
        parts = full.split(sizes)
        batch.latents = torch.cat([t if k is None else t.index_select(0, k) for t, k in zip(parts, batch.img_keep or [None] * len(parts))])
        batch.pixels = None
    if batch.text is None:
        if encode_text is None:
            raise RuntimeError("batch has prompts but no text encoder is bound (set TEXT_ENCODER, or build the text cache)")
        parts = [p.detach().to("cpu") for p in encode_text(batch.prompts)]
        if dataset is not None:
            dataset.write_back(batch, text=parts)
            parts = dataset.texts.as_cached(parts, parts[0].dtype) if dataset.texts.enabled else parts
        set_text(batch, parts)
        batch.prompts = None
    return batch.finalize()


def build_dataset(knobs: dict, text_dim: int | None = None, channels: int | None = None, writer: bool = True, rank: int | None = None):
    """Dataset from the train-script knobs (`DATASETS` entries use `source` or `type`)."""
    return MossDataset(DataConfig.from_knobs(knobs), writer=writer, rank=rank)
