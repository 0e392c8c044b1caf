"""Fold a residual-stream scale into a transformer's weights (the `weights` form of the fp16 fix) and
write it with the factor recorded in the file metadata (`kohakumoss_fp16_fix`); `SCALE=1` undoes a fold.
Role of `scripts/export/fp16_fix.py`. `SCALE="auto"` measures the stream peak on synthetic inputs and
picks the power of two that brings it under TARGET.
"""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
SCALE = "auto"
TARGET = 2048.0
SAVE_DTYPE = "bf16"
OUT = ""
DEVICE = "cpu"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json
    import math

    import torch

    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import resolve_arch
    from kohakumosstrainer_b200.models.io import load_backbone, save_single
    from kohakumosstrainer_b200.models.numerics import SaturationCounter, fold_stream_scale
    from kohakumosstrainer_b200.types.seqinfo import build_seqinfo

    if not OUT:
        raise SystemExit("set OUT")
    arch = resolve_arch(VARIANT, ARCH_OVERRIDES)
    model = build_backbone(arch, device=DEVICE, dtype=torch.float32, seed=0, init=not WEIGHTS).eval()
    if WEIGHTS:
        load_backbone(model, WEIGHTS)
    scale = SCALE
    if scale == "auto":
        counter = SaturationCounter(model)
        seq = build_seqinfo(torch.tensor([[16, 16]]), torch.tensor([32])).to(DEVICE)
        g = torch.Generator().manual_seed(0)
        with torch.no_grad():
            model(torch.randn(seq.n_img, arch.latent_channels, generator=g).to(DEVICE), torch.randn(32, arch.text_dim, generator=g).to(DEVICE),
                  torch.tensor([0.5], device=DEVICE), seq)
        peak = max(counter.peaks.values(), default=1.0)
        scale = 2.0 ** max(0, math.ceil(math.log2(max(peak / float(TARGET), 1.0))))
        print(f"stream peak {peak:.1f}: scale {scale:g}")
    fold_stream_scale(model, float(scale))
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[SAVE_DTYPE]
    save_single(model, OUT, dtype=dtype, metadata={"kohakumoss_fp16_fix": json.dumps({"mode": "weights", "scale": float(scale)})})
    print(f"wrote {OUT}")
    return float(scale)


if __name__ == "__main__":
    main()
