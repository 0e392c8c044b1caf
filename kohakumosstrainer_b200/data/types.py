"""HostBatch: one packed micro-batch in (pinned) host memory.

Fields follow the reference's host batch (`src/kohakumoss_data/types.py:79-117`): packed
latents `[N_img, C]`, packed text embeddings `[N_txt, text_dim]`, latent grids, text lengths
and the `SeqInfo` built on the host. `to_device` ships latents, text and the layout with one
asynchronous copy each from pinned memory and reports the bytes moved.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
from torch import Tensor

from ..types.seqinfo import SeqInfo, build_seqinfo


@dataclass
class HostBatch:
    latents: Tensor | None   # [N_img, C] fp32 / bf16 (None until encoded: `pixels` holds the images)
    text: Tensor | None      # [N_txt, text_dim] (None until encoded: `prompts` holds the captions)
    hw: Tensor               # [B, 2] latent grid per sample
    text_len: Tensor         # [B]
    seq: SeqInfo | None = None
    index: int = 0
    meta: dict = field(default_factory=dict)
    ids: Tensor | None = None            # [B] catalog row ids
    text_drop: Tensor | None = None      # [B] bool: caption dropped this step
    weight: Tensor | None = None         # [B] per-sample loss weight
    img_keep: list | None = None         # per sample: kept image-token indices or None (all)
    pixels: list | None = None           # uint8 [H, W, 3] per sample, when latents are not cached
    prompts: list | None = None          # captions, when text embeddings are not cached
    rank: int = 0
    latent_keys: list = field(default_factory=list)
    text_keys: list = field(default_factory=list)
    text_limit: list = field(default_factory=list)

    def __post_init__(self):
        if self.seq is None and self.latents is not None and self.text is not None:
            self.finalize()

    @property
    def encoded(self) -> bool:
        return self.latents is not None and self.text is not None

    def finalize(self) -> "HostBatch":
        """Build the packed layout once latents, text and `text_len` are known. With
        `img_keep` (image tokens dropped to fit the budget) the layout uses each sample's kept
        positions, so RoPE still sees the original grid coordinates."""
        keep = self.img_keep if self.img_keep and any(k is not None for k in self.img_keep) else None
        self.seq = build_seqinfo(self.hw, self.text_len, img_keep=keep) if keep is not None else build_seqinfo(self.hw, self.text_len)
        return self

    @property
    def samples(self) -> int:
        return int(self.hw.shape[0])

    @property
    def image_tokens(self) -> int:
        return self.seq.n_img

    @property
    def joint_tokens(self) -> int:
        return self.seq.n_joint

    def pin_memory(self) -> "HostBatch":
        if torch.cuda.is_available():
            if self.latents is not None:
                self.latents = self.latents.pin_memory()
            if self.text is not None:
                self.text = self.text.pin_memory()
            if self.seq is not None:
                self.seq.pin_memory()
            if self.weight is not None:
                self.weight = self.weight.pin_memory()
        return self

    def nbytes(self) -> int:
        return (self.latents.numel() * self.latents.element_size() + self.text.numel() * self.text.element_size()
                + self.seq.nbytes())

    def to_device(self, device, latent_dtype=None, text_dtype=None) -> "DeviceBatch":
        z = self.latents.to(device, non_blocking=True)
        t = self.text.to(device, non_blocking=True)
        if latent_dtype is not None:
            z = z.to(latent_dtype)
        if text_dtype is not None:
            t = t.to(text_dtype)
        w = None
        if self.weight is not None and bool((self.weight != 1).any()):
            w = self.weight.to(device, non_blocking=True)
        return DeviceBatch(z, t, self.seq.to(device), self.samples, self.image_tokens, self.nbytes(), w)


@dataclass
class DeviceBatch:
    latents: Tensor
    text: Tensor
    seq: SeqInfo
    samples: int
    image_tokens: int
    h2d_bytes: int = 0
    weight: Tensor | None = None     # [B] per-sample loss weight (None = all ones)
