"""Offline cache passes and the online writer thread.

Offline (`build_latent_cache`, `build_text_cache`): walk what the planner can ask for and
encode whatever the store does not hold yet. For latents that is every live row at its planned
target with the centre crop (and its mirrored twin when `FLIP`); for text every caption
variant of every row plus the dropped caption "". Items are grouped so one encoder call sees
images of one size (`batch` per call). Roles of `src/kohakumoss_data/cache/build.py:1-135`.

Online (`OnlineWriter`): the trainer hands encodings of each step to a queue; one thread per
rank appends them to that rank's shard, so the training loop never waits on the file system
(`src/kohakumoss_data/cache/writer.py:1-180`). `merge_shards` folds the shards back.
"""

from __future__ import annotations

import queue
import threading

import numpy as np
import torch

from .planner import PlanItem, rng_of


def latent_items(dataset) -> list[PlanItem]:
    """Every (row, target, centre crop, flip) the planner can produce for live rows."""
    cat, geo, flips = dataset.catalog, dataset.geometry, (False, True) if dataset.cfg.flip else (False,)
    out = []
    for i in np.nonzero(np.asarray(cat.live, dtype=bool) & (cat.weight > 0))[0].tolist():
        target = tuple(int(v) for v in dataset.planner.targets[i])
        box = geo.center_box(int(cat.w[i]), int(cat.h[i]), target)
        out += [PlanItem(i, target, box, f) for f in flips]
    return out


def build_latent_cache(dataset, encode_images, batch: int = 8, progress=None) -> dict:
    """`encode_images(pixels: list[uint8 HWC tensor], hw [B, 2]) -> [sum(h*w), C]`."""
    store = dataset.latents
    if not store.enabled:
        raise ValueError("LATENT_CACHE is 'off'")
    todo = [(it, store.key(dataset.catalog[it.row_id], it)) for it in latent_items(dataset)]
    todo = [(it, k) for it, k in todo if k not in store.store]
    todo.sort(key=lambda p: p[0].target_hw)
    lf, done = dataset.cfg.latent_factor, 0
    lo = 0
    while lo < len(todo):
        group = [g for g in todo[lo : lo + batch] if g[0].target_hw == todo[lo][0].target_hw]   # sorted: a same-size prefix
        lo += len(group)
        pixels = [torch.from_numpy(dataset.pixels(it)) for it, _ in group]
        hw = torch.tensor([(it.target_hw[0] // lf, it.target_hw[1] // lf) for it, _ in group], dtype=torch.int32)
        full = encode_images(pixels, hw).detach().to("cpu")
        for (it, key), part in zip(group, full.split((hw[:, 0].long() * hw[:, 1].long()).tolist())):
            store.put(key, part)
        done += len(group)
        if progress:
            progress(done, len(todo))
    store.store.close()
    return {"encoded": done, "present": len(store.store)}


def caption_set(dataset) -> list[str]:
    """Every caption the run can ask the text encoder for (deduplicated, "" first when dropout is on)."""
    seen = {"": None} if dataset.cfg.text_drop > 0 else {}
    live = np.nonzero(np.asarray(dataset.catalog.live, dtype=bool))[0].tolist()
    for i in live:
        for v in range(max(1, dataset.cfg.caption_variants)):
            seen.setdefault(dataset.caption(i, v), None)
    return list(seen)


def build_text_cache(dataset, encode_text, batch: int = 16, progress=None) -> dict:
    """`encode_text(prompts) -> list[[L_i, D]]`."""
    store = dataset.texts
    if not store.enabled:
        raise ValueError("TEXT_CACHE is 'off'")
    todo = [(c, store.key(c)) for c in caption_set(dataset)]
    todo = [(c, k) for c, k in todo if k not in store.store]
    todo.sort(key=lambda p: len(p[0]))
    done = 0
    for lo in range(0, len(todo), batch):
        group = todo[lo : lo + batch]
        for (_, key), emb in zip(group, encode_text([c for c, _ in group])):
            store.put(key, emb.detach().to("cpu"))
        done += len(group)
        if progress:
            progress(done, len(todo))
    store.store.close()
    return {"encoded": done, "present": len(store.store)}


class OnlineWriter:
    """Background appends of a step's encodings to this rank's cache shards."""

    def __init__(self, dataset, depth: int = 8):
        self.dataset = dataset
        self.queue: queue.Queue = queue.Queue(depth)
        self.errors: list[str] = []
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self) -> None:
        while True:
            job = self.queue.get()
            if job is None:
                return
            try:
                self.dataset.write_back(*job)
            except Exception as exc:  # a full disk must not kill the training step
                self.errors.append(f"{type(exc).__name__}: {exc}")

    def submit(self, batch, latents=None, text=None) -> bool:
        """Queue a write; a full queue drops it (the sample is simply encoded again later)."""
        try:
            self.queue.put_nowait((batch, None if latents is None else latents.detach().to("cpu"),
                                   None if text is None else [t.detach().to("cpu") for t in text]))
            return True
        except queue.Full:
            return False

    def close(self) -> None:
        self.queue.put(None)
        self.thread.join(timeout=30)
        for cache in (self.dataset.latents, self.dataset.texts):
            if cache.store is not None:
                cache.store.close()
