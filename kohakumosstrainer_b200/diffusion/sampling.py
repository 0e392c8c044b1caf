"""Euler sampling over packed batches: fp32 state and CFG, per-sample seeds and sizes.

CFG modes: `packed` runs cond + uncond samples in ONE packed varlen forward and skips the
negative-branch blocks (block 22 by default) for the uncond segments only; `two_pass` runs two
forwards (`src/kohakumoss/diffusion/sampling/{sample,schedule}.py`). On CUDA the per-step
work (two concatenations, the backbone, the CFG combine and the Euler update) can be captured
once into a CUDA graph and replayed for every sigma (`graph=True`): the sampler loop is
launch-bound at small batch.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass

import torch
from torch import Tensor

from ..types.seqinfo import SeqInfo, build_seqinfo
from .timestep import shift_sigma

LATENT_FACTOR = 16  # pixels per latent token side: VAE /8 times the 2x2 patchify
Size = tuple[int, int]


@dataclass
class SampleResult:
    latents: Tensor  # packed [N_img, C]
    hw: Tensor  # [B, 2]

    def per_image(self) -> list[Tensor]:
        """The packed latents split per image: `[h * w, C]` each."""
        sizes = (self.hw[:, 0].long() * self.hw[:, 1].long()).tolist()
        return list(self.latents.split(sizes, 0))


def moss_sigmas(steps: int = 50, shift: float = 5.0, total: int = 1000, training_shift: float = 1.0) -> Tensor:
    """Descending fp32 sigmas ending in 0: `steps` shifted values snapped to the nearest
    training-grid sigma, consecutive duplicates dropped."""
    if steps < 1 or shift <= 0 or training_shift <= 0:
        raise ValueError("steps and shifts must be positive")

    def grid(count, s):
        lower = s / (total + s - 1)
        return shift_sigma(torch.linspace(1, lower, count, dtype=torch.float32), s)

    sigmas = grid(steps, shift)
    training = grid(total, training_shift).flip(0)
    upper = torch.searchsorted(training, sigmas).clamp(max=total - 1)
    lower = (upper - 1).clamp(min=0)
    nearer_lower = (sigmas - training[lower]).abs() <= (training[upper] - sigmas).abs()
    snapped = torch.unique_consecutive(training[torch.where(nearer_lower, lower, upper)])
    return torch.cat((snapped, snapped.new_zeros(1)))


def latent_grid(sizes: Size | Sequence[Size], count: int) -> Tensor:
    if isinstance(sizes[0], int):
        sizes = [sizes] * count
    if len(sizes) != count:
        raise ValueError(f"{len(sizes)} sizes for {count} samples")
    for h, w in sizes:
        if h <= 0 or w <= 0 or h % LATENT_FACTOR or w % LATENT_FACTOR:
            raise ValueError(f"size {(h, w)} must be positive multiples of {LATENT_FACTOR}")
    return torch.tensor([[h // LATENT_FACTOR, w // LATENT_FACTOR] for h, w in sizes])


def initial_noise(seeds: Sequence[int], hw: Tensor, channels: int, device) -> Tensor:
    """Packed fp32 noise; sample i depends only on (seeds[i], hw[i])."""
    out = []
    for seed, (h, w) in zip(seeds, hw.tolist()):
        g = torch.Generator(device).manual_seed(int(seed))
        z = torch.randn((1, channels, h, w), generator=g, device=device)
        out.append(z[0].flatten(1).transpose(0, 1))
    return torch.cat(out)


def unpack(latents: Tensor, hw: Tensor) -> list[Tensor]:
    out, start = [], 0
    for h, w in hw.tolist():
        n = h * w
        out.append(latents[start : start + n].transpose(0, 1).reshape(1, -1, h, w))
        start += n
    return out


def _cat(text: Sequence[Tensor], device) -> tuple[Tensor, Tensor]:
    return torch.cat([t.to(device) for t in text]), torch.tensor([t.shape[0] for t in text])


def _layout(hw: Tensor, text_len: Tensor, device) -> SeqInfo:
    with torch.inference_mode(False):
        return build_seqinfo(hw, text_len).to(device)


def build_velocity(backbone, hw, positive, negative, cfg: float, skip: frozenset, device, cfg_mode: str) -> Callable:
    """`velocity(x fp32 [N_img, C], sigma [B]) -> v fp32` for the chosen CFG mode."""
    dtype = backbone.compute_dtype()
    if cfg == 1.0 or negative is None:
        text, lens = _cat(positive, device)
        seq = _layout(hw, lens, device)
        forward = backbone.bind_forward()
        text = text.to(dtype)
        return lambda x, s: forward(x.to(dtype), text, s, seq).float()
    pos_text, pos_len = _cat(positive, device)
    neg_text, neg_len = _cat(negative, device)
    if cfg_mode == "two_pass":
        pos_seq, neg_seq = _layout(hw, pos_len, device), _layout(hw, neg_len, device)
        cond, uncond = backbone.bind_forward(), backbone.bind_forward(tuple(sorted(skip)))
        pos_text, neg_text = pos_text.to(dtype), neg_text.to(dtype)

        def velocity(x, s):
            v = cond(x.to(dtype), pos_text, s, pos_seq).float()
            u = uncond(x.to(dtype), neg_text, s, neg_seq).float()
            return u + cfg * (v - u)

        return velocity
    if cfg_mode != "packed":
        raise ValueError(f"CFG_MODE must be packed|two_pass, got {cfg_mode}")
    b = hw.shape[0]
    text = torch.cat((pos_text, neg_text)).to(dtype)
    seq = _layout(torch.cat((hw, hw)), torch.cat((pos_len, neg_len)), device)
    uncond_mask = torch.arange(2 * b, device=device) >= b
    forward = backbone.bind_forward(segment_skip_layers=tuple(sorted(skip))) if skip else None
    plain = backbone.bind_forward()

    def velocity(x, s):
        n = x.shape[0]
        xx = torch.cat((x, x)).to(dtype)
        ss = torch.cat((s, s))
        out = (forward(xx, text, ss, seq, uncond_mask) if forward is not None else plain(xx, text, ss, seq)).float()
        v, u = out[:n], out[n:]
        return u + cfg * (v - u)

    return velocity


@torch.no_grad()
def sample_latents(
    backbone,
    positive: Sequence[Tensor],
    negative: Sequence[Tensor] | None,
    size: Size | Sequence[Size] = (1024, 1024),
    steps: int = 50,
    cfg: float = 3.0,
    shift: float = 5.0,
    skip_layers: Sequence[int] | None = None,
    seeds: Sequence[int] = (0,),
    device="cuda",
    cfg_mode: str = "packed",
    callback: Callable[[int, Tensor], None] | None = None,
    noise: Tensor | None = None,
    graph: bool = False,
) -> SampleResult:
    """Euler integration of the velocity field from sigma = 1 to 0.

    `positive` / `negative`: per-sample unpadded text embeddings `[L_i, text_dim]`; `cfg == 1`
    runs the positive branch only. `skip_layers=None` uses the architecture's negative-skip
    blocks; indices outside `[0, depth)` raise."""
    b = len(positive)
    if len(seeds) != b:
        raise ValueError("one seed per sample")
    hw = latent_grid(size, b)
    if skip_layers is None:
        skip_layers = backbone.cfg.negative_skip_layers
    depth = backbone.cfg.depth
    outside = sorted(i for i in skip_layers if not 0 <= i < depth)
    if outside:
        raise ValueError(f"skip layers {outside} outside the {depth} blocks")
    velocity = build_velocity(backbone, hw, positive, negative, cfg, frozenset(skip_layers), device, cfg_mode)
    x = initial_noise(seeds, hw, backbone.cfg.latent_channels, device) if noise is None else noise.to(device, torch.float32)
    sigmas = moss_sigmas(steps, shift).to(device)
    n_steps = len(sigmas) - 1
    if graph and torch.device(device).type == "cuda" and n_steps > 2:
        x = _graphed_loop(velocity, x, sigmas, b, callback)
        return SampleResult(x, hw)
    for i in range(n_steps):
        v = velocity(x, sigmas[i].expand(b))
        x = x + (sigmas[i + 1] - sigmas[i]) * v
        if callback is not None:
            callback(i, x)
    return SampleResult(x, hw)


def _graphed_loop(velocity, x, sigmas, b, callback):
    """Capture one Euler step (static buffers for x, sigma, d sigma) and replay it."""
    static_x = x.clone()
    sig = torch.zeros(b, device=x.device)
    dsig = torch.zeros((), device=x.device)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(2):  # warm-up outside capture: lazy allocations, packs, tables
            sig.copy_(sigmas[i].expand(b))
            velocity(static_x, sig)
    torch.cuda.current_stream().wait_stream(stream)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        v = velocity(static_x, sig)
        static_x.add_(dsig * v)
    for i in range(len(sigmas) - 1):
        sig.copy_(sigmas[i].expand(b))
        dsig.copy_(sigmas[i + 1] - sigmas[i])
        g.replay()
        if callback is not None:
            callback(i, static_x)
    return static_x.clone()
