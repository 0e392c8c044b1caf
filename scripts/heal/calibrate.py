"""Report the massive channels of a model: per-channel peak RMS ratio over the reader-norm sites
and the shrink each TAU would apply (role of `scripts/heal/calibrate.py`)."""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
DATASETS = [{"type": "synthetic"}]
MAX_TOKENS = 8192
SIZE_STEP = 64
SEED = 0
TAUS = (4.0, 8.0, 16.0)
CALIB_BATCHES = 8
OUT = ""
DEVICE = "cuda"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json

    import torch

    from kohakumosstrainer_b200.config import collect
    from kohakumosstrainer_b200.heal import Heal, HealConfig, shrink_scales, top_channels
    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import resolve_arch
    from kohakumosstrainer_b200.models.io import load_backbone
    from kohakumosstrainer_b200.training.entry import build_dataset

    k = collect(globals())
    device = torch.device(DEVICE if torch.cuda.is_available() else "cpu")
    dtype = torch.float32 if device.type == "cpu" else torch.bfloat16
    arch = resolve_arch(VARIANT, ARCH_OVERRIDES)
    model = build_backbone(arch, device=device, dtype=dtype, seed=SEED, init=not WEIGHTS)
    if WEIGHTS:
        load_backbone(model, WEIGHTS)
    heal = Heal(model, HealConfig(tau=max(TAUS), steps=0, calib_batches=CALIB_BATCHES, seed=SEED), build_dataset({**k, "SIZE_STEP": SIZE_STEP}, arch.text_dim, arch.latent_channels),
                device, dtype)
    peak = heal.report["peak"]
    report = {"top": top_channels(peak, 32), "taus": {str(t): int((shrink_scales(peak, t) < 1).sum()) for t in TAUS}}
    print(json.dumps(report, indent=1))
    if OUT:
        with open(OUT, "w", encoding="utf-8") as f:
            json.dump(report, f, indent=1)
    return report


if __name__ == "__main__":
    main()
