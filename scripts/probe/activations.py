"""Residual-stream statistics per block on synthetic (or cached) batches: RMS, peak, top-8 channel energy share and
the channels with the largest peak ratio (role of `scripts/probe/activations.py`).

    python -m kohakumosstrainer_b200.cli.run scripts/probe/activations.py --set WEIGHTS=<model>
"""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
MAX_TOKENS = 4096
BATCHES = 2
SIGMA = 0.5
DEVICE = "cuda"
OUT = ""

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json

    import torch

    from kohakumosstrainer_b200.data import SyntheticConfig, SyntheticDataset
    from kohakumosstrainer_b200.diffusion.objective import noise_latents
    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import resolve_arch
    from kohakumosstrainer_b200.models.io import load_backbone
    from kohakumosstrainer_b200.training.extras import top_share

    device = torch.device(DEVICE if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    arch = resolve_arch(VARIANT, ARCH_OVERRIDES)
    model = build_backbone(arch, device=device, dtype=dtype, seed=0, init=not WEIGHTS).eval()
    if WEIGHTS:
        load_backbone(model, WEIGHTS)
    stats = {i: {"rms": 0.0, "peak": 0.0, "top8": 0.0} for i in range(arch.depth)}

    def hook(i):
        def fn(m, a, out):
            s = stats[i]
            s["rms"] += float(out.float().square().mean().sqrt()) / BATCHES
            s["peak"] = max(s["peak"], float(out.abs().max()))
            s["top8"] += float(top_share(out, 8)) / BATCHES
        return fn

    for i, layer in enumerate(model.layers):
        layer.register_forward_hook(hook(i))
    data = SyntheticDataset(SyntheticConfig(max_tokens=int(MAX_TOKENS), min_area=256 * 256, max_area=512 * 512, channels=arch.latent_channels,
                                            text_dim=arch.text_dim, dtype=torch.float32))
    g = torch.Generator(device).manual_seed(0)
    with torch.no_grad():
        for i in range(int(BATCHES)):
            b = data.materialize(i).to_device(device, torch.float32, dtype)
            sigma = torch.full((b.seq.batch,), float(SIGMA), device=device)
            eps = torch.randn(b.latents.shape, generator=g, device=device)
            z, _ = noise_latents(b.latents.float(), eps, sigma, b.seq.seg_img)
            model(z.to(dtype), b.text.to(dtype), sigma, b.seq)
    for i, s in stats.items():
        print(f"block {i:2d}: rms {s['rms']:.4g} peak {s['peak']:.4g} top8 share {s['top8']:.3f}")
    if OUT:
        with open(OUT, "w", encoding="utf-8") as f:
            json.dump(stats, f, indent=1)
    return stats


if __name__ == "__main__":
    main()
