"""Comparison grid: the same prompts and seeds sampled under several settings (adapters on / off, multipliers,
CFG values, step counts), written side by side: one folder per column plus `grid.json`, and a PNG contact sheet
when a VAE is bound (role of `scripts/sample/compare_grid.py`). Without encoders it runs on synthetic embeddings
and writes latents.

    python -m kohakumosstrainer_b200.cli.run scripts/sample/compare_grid.py --set COLUMNS="[{'cfg': 1.0}, {'cfg': 3.0}, {'cfg': 5.0}]"
"""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
PRECISION = "bf16"
BASE_PRECISION = "auto"
FP8_RECIPE = "row"
PROMPTS = ["a photo of a cat"]
NEGATIVE = ""
SEEDS = (0,)
SIZE = (1024, 1024)
STEPS = 32
CFG = 3.0
SHIFT = 5.0
COLUMNS = [{}]          # per column: overrides among cfg, steps, shift, adapters [(path, multiplier)], skip_layers
OUT = "outputs/grid"
DEVICE = "cuda"
TEXT_DIM_TOKENS = 64

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json
    from pathlib import Path

    import torch

    from kohakumosstrainer_b200.diffusion.sampling import sample_latents
    from kohakumosstrainer_b200.encoders import synthetic_text_encoder
    from kohakumosstrainer_b200.inference import MossPipeline

    device = DEVICE if torch.cuda.is_available() else "cpu"
    out = Path(OUT)
    out.mkdir(parents=True, exist_ok=True)
    record = []
    for c, col in enumerate(COLUMNS):
        pipe = MossPipeline.from_pretrained(WEIGHTS, VARIANT, dict(ARCH_OVERRIDES), device=device, precision=PRECISION, base_precision=BASE_PRECISION,
                                            fp8_recipe=FP8_RECIPE, adapters=list(col.get("adapters", [])))
        arch = pipe.backbone.cfg
        enc = synthetic_text_encoder(arch.text_dim)
        pos = [p.to(pipe.device, pipe.dtype) for p in enc(PROMPTS)]
        neg = [p.to(pipe.device, pipe.dtype) for p in enc([NEGATIVE] * len(PROMPTS))]
        folder = out / f"col{c:02d}"
        folder.mkdir(exist_ok=True)
        for seed in SEEDS:
            res = sample_latents(pipe.backbone, pos, neg, size=tuple(SIZE), steps=int(col.get("steps", STEPS)), cfg=float(col.get("cfg", CFG)),
                                 shift=float(col.get("shift", SHIFT)), skip_layers=col.get("skip_layers"), seeds=[seed] * len(pos), device=pipe.device)
            for i, z in enumerate(res.per_image()):
                torch.save(z.cpu(), folder / f"{i}_{seed}.pt")
        record.append({"column": c, "settings": {k: v for k, v in col.items()}, "folder": str(folder)})
        del pipe
    (out / "grid.json").write_text(json.dumps({"prompts": PROMPTS, "seeds": list(SEEDS), "columns": record}, indent=1))
    print(f"wrote {len(COLUMNS)} columns to {out}")
    return record


if __name__ == "__main__":
    main()
