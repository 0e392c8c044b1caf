"""Sampling trajectory probe: per Euler step the latent RMS, the velocity RMS and the cosine between consecutive
velocities, for one prompt and seed (role of `scripts/probe/trajectory.py`)."""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
SIZE = (512, 512)
STEPS = 16
CFG = 3.0
SEED = 0
DEVICE = "cuda"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import torch

    from kohakumosstrainer_b200.diffusion.sampling import sample_latents
    from kohakumosstrainer_b200.encoders import synthetic_text_encoder
    from kohakumosstrainer_b200.inference import MossPipeline

    device = DEVICE if torch.cuda.is_available() else "cpu"
    pipe = MossPipeline.from_pretrained(WEIGHTS, VARIANT, dict(ARCH_OVERRIDES), device=device)
    enc = synthetic_text_encoder(pipe.backbone.cfg.text_dim)
    pos = [p.to(pipe.device, pipe.dtype) for p in enc(["a probe prompt"])]
    neg = [p.to(pipe.device, pipe.dtype) for p in enc([""])]
    rows, prev = [], {"x": None, "v": None}

    def cb(i, x):
        if prev["x"] is not None:
            v = x - prev["x"]
            cos = float(torch.nn.functional.cosine_similarity(v.flatten(), prev["v"].flatten(), dim=0)) if prev["v"] is not None else float("nan")
            rows.append({"step": i, "latent_rms": float(x.square().mean().sqrt()), "delta_rms": float(v.square().mean().sqrt()), "cos_prev": cos})
            prev["v"] = v
        prev["x"] = x.clone()

    sample_latents(pipe.backbone, pos, neg, size=tuple(SIZE), steps=int(STEPS), cfg=float(CFG), seeds=[int(SEED)], device=pipe.device, callback=cb)
    for r in rows:
        print(r)
    return rows


if __name__ == "__main__":
    main()
