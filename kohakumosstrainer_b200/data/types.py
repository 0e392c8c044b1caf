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
    latents: Tensor          # [N_img, C] fp32 / bf16
    text: Tensor             # [N_txt, text_dim]
    hw: Tensor               # [B, 2] latent grid per sample
    text_len: Tensor         # [B]
    seq: SeqInfo | None = None
    index: int = 0
    meta: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.seq is None:
            self.seq = build_seqinfo(self.hw, self.text_len)

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
            self.latents = self.latents.pin_memory()
            self.text = self.text.pin_memory()
            self.seq.pin_memory()
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
        return DeviceBatch(z, t, self.seq.to(device), self.samples, self.image_tokens, self.nbytes())


@dataclass
class DeviceBatch:
    latents: Tensor
    text: Tensor
    seq: SeqInfo
    samples: int
    image_tokens: int
    h2d_bytes: int = 0
