"""Optional encoders around the DiT: the Qwen text encoder and the FLUX.2 VAE.

Neither model ships with this repository and neither `diffusers` nor the weights are available
offline, so both are thin, lazily imported wrappers with the reference's interface
(`src/kohakumoss/encoders/text/encoder.py`, `encoders/vae/__init__.py`): `encode(prompts) ->
list[[L_i, 4096]]` and `encode(images) / decode(latents)` with the 32-channel /8 latent
patchified 2 x 2 into 128 channels and normalised by running statistics. Training and sampling
entry points accept ready text embeddings and latents, which is what the caches of the data
layer store.
"""

from __future__ import annotations

import torch
from torch import Tensor


class QwenTextEncoder:
    """`transformers` causal LM used as an embedding model: last hidden state per prompt,
    unpadded."""

    def __init__(self, path: str, device="cuda", dtype=torch.bfloat16, max_tokens: int = 4096):
        from transformers import AutoModel, AutoTokenizer

        self.tokenizer = AutoTokenizer.from_pretrained(path)
        self.model = AutoModel.from_pretrained(path, torch_dtype=dtype).to(device).eval()
        self.device, self.max_tokens = torch.device(device), max_tokens

    @torch.no_grad()
    def encode(self, prompts: list[str]) -> list[Tensor]:
        out = []
        for text in prompts:
            ids = self.tokenizer(text, return_tensors="pt", truncation=True, max_length=self.max_tokens).to(self.device)
            out.append(self.model(**ids).last_hidden_state[0])
        return out


def patchify(z: Tensor) -> Tensor:
    """[B, 32, H, W] -> [B, 128, H/2, W/2] (2 x 2 patches into channels)."""
    b, c, h, w = z.shape
    return z.reshape(b, c, h // 2, 2, w // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(b, c * 4, h // 2, w // 2)


def unpatchify(z: Tensor) -> Tensor:
    b, c, h, w = z.shape
    return z.reshape(b, c // 4, 2, 2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(b, c // 4, h * 2, w * 2)


class FluxVae:
    """Wrapper of a diffusers `AutoencoderKL`-style FLUX.2 VAE (needs `diffusers`)."""

    def __init__(self, path: str, device="cuda", dtype=torch.bfloat16, mean: Tensor | None = None, std: Tensor | None = None):
        try:
            from diffusers import AutoencoderKL
        except ImportError as err:  # pragma: no cover - not installed on the build image
            raise RuntimeError("the VAE wrapper needs the `diffusers` package") from err
        self.vae = AutoencoderKL.from_pretrained(path, torch_dtype=dtype).to(device).eval()
        self.mean = mean if mean is not None else torch.zeros(128)
        self.std = std if std is not None else torch.ones(128)

    @torch.no_grad()
    def encode(self, images: Tensor) -> Tensor:
        z = patchify(self.vae.encode(images).latent_dist.mode())
        return (z - self.mean.to(z)[None, :, None, None]) / self.std.to(z)[None, :, None, None]

    @torch.no_grad()
    def decode(self, latents: Tensor):
        z = latents * self.std.to(latents)[None, :, None, None] + self.mean.to(latents)[None, :, None, None]
        return self.vae.decode(unpatchify(z)).sample
