"""Target sizes and crop boxes.

Sizes are `(h, w)` pixels, multiples of `step`; crop boxes are `(l, t, r, b)` source pixels
with the target's aspect (crop first, then resize). One latent token covers
`latent_factor` x `latent_factor` pixels (VAE /8 times the 2 x 2 patchify). Behaviour
follows the reference geometry (`src/kohakumoss_data/resolution/geometry.py:14-118`); the
row-wise fit here is vectorised over the whole catalog (`fit_many`).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

LATENT_FACTOR = 16


@dataclass(frozen=True)
class Geometry:
    area: int = 1024 * 1024
    step: int = LATENT_FACTOR
    aspect_range: tuple[float, float] = (0.25, 4.0)
    upscale: str = "never"          # never | to_area
    crop: str = "center"            # center | random
    latent_factor: int = LATENT_FACTOR

    def __post_init__(self):
        if self.step % self.latent_factor:
            raise ValueError("step must be a multiple of latent_factor")
        if self.upscale not in ("never", "to_area"):
            raise ValueError(f"upscale must be never|to_area, got {self.upscale}")
        if self.crop not in ("center", "random"):
            raise ValueError(f"crop must be center|random, got {self.crop}")

    # -- token counts -----------------------------------------------------------------------
    def tokens(self, hw) -> int:
        return (int(hw[0]) // self.latent_factor) * (int(hw[1]) // self.latent_factor)

    def tokens_many(self, hw: np.ndarray) -> np.ndarray:
        return (hw[:, 0] // self.latent_factor) * (hw[:, 1] // self.latent_factor)

    # -- native-aspect fit --------------------------------------------------------------------
    def clamp_aspect(self, w: int, h: int) -> tuple[int, int]:
        """Largest centred sub-size of (w, h) whose aspect w/h lies in `aspect_range`."""
        lo, hi = self.aspect_range
        a = w / h
        if a > hi:
            return max(1, round(h * hi)), h
        if a < lo:
            return w, max(1, round(w / lo))
        return w, h

    def fit(self, w: int, h: int, area: int | None = None) -> tuple[int, int]:
        """Target (h, w) of at most `area` pixels with the (clamped) source aspect."""
        area = area or self.area
        cw, ch = self.clamp_aspect(w, h)
        scale = math.sqrt(area / (cw * ch))
        if self.upscale == "never":
            scale = min(scale, 1.0)
        s = self.step
        tw = max(s, int(cw * scale) // s * s)
        th = max(s, int(ch * scale) // s * s)
        want = math.log(cw / ch)
        best = None
        for ch_, cw_ in ((th, tw), (th - s, tw), (th, tw - s)):
            if ch_ < s or cw_ < s:
                continue
            err = abs(math.log(cw_ / ch_) - want)
            if best is None or err < best[0]:
                best = (err, ch_, cw_)
        _, th, tw = best
        lo, hi = self.aspect_range
        while tw / th > hi and tw > s:
            tw -= s
        while tw / th < lo and th > s:
            th -= s
        return th, tw

    def fit_many(self, w: np.ndarray, h: np.ndarray) -> np.ndarray:
        """`fit` for every row: int64 [N, 2] of (h, w). Rows sharing a size share the result."""
        pairs = np.stack([np.asarray(w, dtype=np.int64), np.asarray(h, dtype=np.int64)], 1)
        uniq, inverse = np.unique(pairs, axis=0, return_inverse=True)
        fitted = np.array([self.fit(int(a), int(b)) for a, b in uniq], dtype=np.int64).reshape(-1, 2)
        return fitted[inverse.reshape(-1)]

    # -- fixed shapes -------------------------------------------------------------------------
    def square(self) -> int:
        return max(self.step, int(math.sqrt(self.area)) // self.step * self.step)

    def buckets(self) -> list[tuple[int, int]]:
        """(h, w) buckets of about `area` pixels across the aspect range, one per width step."""
        lo, hi = self.aspect_range
        out = set()
        w = self.step
        limit = math.sqrt(self.area * hi) + self.step
        while w <= limit:
            h = int(self.area / w) // self.step * self.step
            if h >= self.step and lo <= w / h <= hi:
                out.add((h, w))
            w += self.step
        return sorted(out, key=lambda hw: hw[1] / hw[0])

    # -- crop boxes ---------------------------------------------------------------------------
    def box_size(self, w: int, h: int, target) -> tuple[int, int]:
        th, tw = target
        a = tw / th
        if w / h > a:
            return max(1, min(w, round(h * a))), h
        return w, max(1, min(h, round(w / a)))

    def center_box(self, w: int, h: int, target, rng=None) -> tuple[int, int, int, int]:
        cw, ch = self.box_size(w, h, target)
        left, top = (w - cw) // 2, (h - ch) // 2
        return left, top, left + cw, top + ch

    def random_box(self, w: int, h: int, target, rng) -> tuple[int, int, int, int]:
        cw, ch = self.box_size(w, h, target)
        left = int(rng.integers(0, w - cw + 1))
        top = int(rng.integers(0, h - ch + 1))
        return left, top, left + cw, top + ch

    def box(self, w: int, h: int, target, rng) -> tuple[int, int, int, int]:
        return self.random_box(w, h, target, rng) if self.crop == "random" else self.center_box(w, h, target, rng)


def nearest_bucket(w: int, h: int, buckets) -> tuple[int, int]:
    """The (h, w) bucket whose log aspect is closest to w / h."""
    want = math.log(w / h)
    return min(buckets, key=lambda hw: abs(math.log(hw[1] / hw[0]) - want))


def nearest_bucket_many(w: np.ndarray, h: np.ndarray, buckets) -> np.ndarray:
    """Index into `buckets` per row (vectorised `nearest_bucket`)."""
    b = np.asarray(buckets, dtype=np.float64)
    logs = np.log(b[:, 1] / b[:, 0])
    want = np.log(np.asarray(w, dtype=np.float64) / np.asarray(h, dtype=np.float64))
    return np.abs(want[:, None] - logs[None, :]).argmin(1)
