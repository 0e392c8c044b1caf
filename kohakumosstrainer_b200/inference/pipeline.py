"""MossPipeline: DiT + (optional) text encoder and VAE -> images or latents.

`from_pretrained` builds the DiT (checkpoint or random init), applies the base precision
(fp8 per-tensor / row compute), attaches adapters (merged or bypass) and places the optional
encoders; `generate` encodes prompts (or takes ready text embeddings), samples in chunks of
`batch` with packed CFG and the negative-branch block skip, and decodes when a VAE is present
(`src/kohakumoss/inference/pipeline.py:177-494` in the reference). New here: the Euler step is
replayed from a CUDA graph, and `generate_distributed` shards the requests over the ranks of a
process group (data-parallel sampling, no communication except gathering timings).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path

import torch
from torch import Tensor

from ..diffusion.sampling import sample_latents, unpack
from ..models import build_backbone
from ..models.build import resolve_arch
from ..quant import apply_base_precision


@dataclass
class SampleRequest:
    positive: Tensor                 # [L, text_dim] text embedding (or produced from `prompt`)
    negative: Tensor | None = None
    size: tuple[int, int] = (1024, 1024)
    seed: int = 0
    prompt: str = ""
    meta: dict = field(default_factory=dict)


def batch_slices(n: int, batch: int):
    for start in range(0, n, max(1, batch)):
        yield slice(start, min(n, start + batch))


class MossPipeline:
    def __init__(self, backbone, text_encoder=None, vae=None, device="cuda", dtype=torch.bfloat16):
        self.backbone, self.text_encoder, self.vae = backbone, text_encoder, vae
        self.device, self.dtype = torch.device(device), dtype
        self.step_log: list[dict] = []

    @classmethod
    def from_pretrained(cls, weights: str = "", variant: str = "base", arch_overrides: dict | None = None, device="cuda",
                        precision: str = "bf16", base_precision: str = "auto", fp8_recipe: str = "row",
                        adapters: list[tuple[str, float]] | None = None, adapter_mode: str = "merge",
                        text_encoder=None, vae=None, seed: int = 0, kernels: dict | None = None) -> "MossPipeline":
        dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16, "auto": torch.bfloat16}[precision]
        device = torch.device(device)
        if device.type == "cpu":
            dtype = torch.float32
        arch = resolve_arch(variant, arch_overrides)
        transformer = weights
        if weights and Path(weights).is_dir() and (Path(weights) / "transformer").is_dir():
            transformer = str(Path(weights) / "transformer")  # HF pipeline folder layout
        if transformer and Path(transformer).is_dir():
            from ..models.io import arch_from_config

            arch = arch_from_config(transformer) or arch
        model = build_backbone(arch, device=device, dtype=dtype, seed=seed, init=not transformer)
        if transformer:
            from ..models.io import load_backbone

            load_backbone(model, transformer)
        if kernels:
            from ..ops import resolve_ops

            model.bind_ops(resolve_ops(device, kernels))
        merged_first = adapter_mode == "merge"
        if adapters and merged_first:
            cls._attach(model, adapters, "merge")
            cls._fold_merged(model)
        apply_base_precision(model, base_precision, fp8_recipe)
        if adapters and not merged_first:
            cls._attach(model, adapters, "bypass")
        for p in model.parameters():
            p.requires_grad_(False)
        model.eval()
        return cls(model, text_encoder, vae, device, dtype)

    @staticmethod
    def _use_graph(graph, chunk, steps) -> bool:
        """`graph="auto"`: capture the sampler step only where launches dominate: few packed tokens per step (a capture
        costs about one eager step, and at 4 x 1024^2 with CFG the step is ~0.33 s of kernels, not launches)."""
        if graph != "auto":
            return bool(graph)
        tokens = 2 * sum((r.size[0] // 16) * (r.size[1] // 16) for r in chunk)
        return tokens <= 4096 and steps >= 8

    @staticmethod
    def _attach(model, adapters, mode):
        from ..adapters.export import load_adapters

        for path, mult in adapters:
            load_adapters(model, path, multiplier=mult, mode=mode)

    @staticmethod
    def _fold_merged(model) -> None:
        """Write W + dW into the dense weights and drop the adapter modules."""
        from ..models.linear import MossLinear

        with torch.no_grad():
            for m in model.modules():
                if isinstance(m, MossLinear) and m.adapter is not None:
                    m.weight.copy_(m.effective_weight(torch.float32).to(m.weight.dtype))
                    m.set_adapter(None)

    # -- encode ----------------------------------------------------------------------------
    def encode(self, prompts: list[str]) -> list[Tensor]:
        if self.text_encoder is None:
            raise RuntimeError("no text encoder attached: pass text embeddings in the requests")
        return self.text_encoder.encode(prompts)

    # -- sample ----------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, requests: list[SampleRequest], steps: int = 50, cfg: float = 3.0, shift: float = 5.0,
                 skip_layers="default", cfg_mode: str = "packed", batch: int = 4, graph: bool | str = "auto", decode: bool = True) -> dict:
        """Returns {"latents": [ [1, C, h, w] ... ], "images": [...] or None, "seconds": wall,
        "device_ms": device time of the sampling loops, "per_image_s": device seconds / image}."""
        if skip_layers == "default":
            skip = None
        elif skip_layers in ("none", None, ()):
            skip = ()
        else:
            skip = tuple(int(s) for s in (skip_layers.split(",") if isinstance(skip_layers, str) else skip_layers))
        latents, device_ms = [], 0.0
        t0 = time.perf_counter()
        for sl in batch_slices(len(requests), batch):
            chunk = requests[sl]
            pos = [r.positive.to(self.device) for r in chunk]
            neg = None
            if cfg != 1.0:
                neg = [(r.negative if r.negative is not None else torch.zeros_like(r.positive[:1])).to(self.device) for r in chunk]
            cuda = self.device.type == "cuda"
            if cuda:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            res = sample_latents(self.backbone, pos, neg, [r.size for r in chunk], steps, cfg, shift, skip,
                                 [r.seed for r in chunk], self.device, cfg_mode, graph=self._use_graph(graph, chunk, steps) and cuda)
            if cuda:
                end.record()
                end.synchronize()
                device_ms += start.elapsed_time(end)
            latents += unpack(res.latents, res.hw)
            self.step_log.append({"images": len(chunk), "steps": steps})
        images = None
        if decode and self.vae is not None:
            images = [self.vae.decode(z) for z in latents]
        wall = time.perf_counter() - t0
        n = max(1, len(requests))
        return {"latents": latents, "images": images, "seconds": wall, "device_ms": device_ms,
                "per_image_s": (device_ms / 1e3 if device_ms else wall) / n}

    def generate_distributed(self, requests: list[SampleRequest], rank: int, world: int, **kw) -> dict:
        """Data-parallel sampling: rank r takes requests r, r + world, ...; results stay local."""
        mine = requests[rank::world]
        out = self.generate(mine, **kw)
        out["indices"] = list(range(rank, len(requests), world))
        return out


def synthetic_requests(n: int, text_dim: int, size=(1024, 1024), text_tokens: int = 256, seed: int = 0, dtype=torch.bfloat16):
    """N(0, 1) text embeddings standing in for encoder output (benchmarks and tests)."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for i in range(n):
        pos = torch.randn(text_tokens, text_dim, generator=g).to(dtype)
        neg = torch.randn(text_tokens, text_dim, generator=g).to(dtype)
        out.append(SampleRequest(pos, neg, size, seed=seed + i))
    return out
